"""ctypes signatures and argument blocks of the peer-to-peer / multimem communication kernels
(csrc/comm_p2p.cu). The structures mirror `ArSgdArgs`, `MixArgs` and `BarrierArgs` field by field."""
import ctypes as C

vp, i32, i64, f32, u32 = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_uint
MAX_RANKS = 8

SIGS = {
    "rb_allreduce_sgd_p2p": [vp, i32, vp],
    "rb_allreduce_push_p2p": [vp, i32, vp],
    "rb_allreduce_wait_p2p": [vp, vp],
    "rb_publish_p2p": [vp, i32, vp],
    "rb_gossip_mix_p2p": [vp, i32, vp],
    "rb_push_add_p2p": [vp, i32, vp],
    "rb_push_finalize": [vp, i32, vp],
    "rb_elastic_pull_p2p": [vp, i32, vp],
    "rb_elastic_apply": [vp, vp, i64, vp],
    "rb_push_begin_p2p": [vp, vp],
    "rb_push_add_async_p2p": [vp, i32, vp],
    "rb_fold_begin_p2p": [vp, vp],
    "rb_fold_p2p": [vp, i32, vp],
    "rb_elastic_begin_p2p": [vp, vp],
    "rb_elastic_mix_p2p": [vp, i32, vp],
    "rb_barrier_p2p": [vp, vp],
    "rb_link_probe": [vp, vp, vp, i64, i32, i32, i32, i32, vp],
}


class SgdHyper(C.Structure):
    _fields_ = [("lr", f32), ("mu", f32), ("l2", f32), ("grad_scale", f32), ("mode", i32), ("phase", i32)]


class ArSgdArgs(C.Structure):
    _fields_ = [("grads", vp * MAX_RANKS), ("w16", vp * MAX_RANKS), ("w32", vp * MAX_RANKS),
                ("flags", vp * MAX_RANKS), ("stage", vp * MAX_RANKS), ("w", vp), ("v", vp), ("mc_grads", vp),
                ("mc_w16", vp), ("epoch_ptr", vp), ("block_counter", vp), ("status", vp), ("wait_ok", vp), ("off", i64),
                ("n", i64), ("decay_len", i64), ("stage_off", i64), ("rank", i32), ("world", i32), ("slot", i32),
                ("one_shot", i32), ("op", i32), ("zero_grads", i32), ("avg_scale", f32), ("h", SgdHyper), ("wait_ns", i64)]


class MixArgs(C.Structure):
    _fields_ = [("flags", vp * MAX_RANKS), ("w", vp), ("w16", vp), ("pub_local", vp), ("pub_peer", vp),
                ("acc_target", vp), ("count_target", vp), ("epoch_ptr", vp), ("block_counter", vp), ("status", vp),
                ("n", i64), ("rank", i32), ("world", i32), ("slot", i32), ("peer", i32), ("wait_peer", i32),
                ("alpha", f32), ("w_self", f32), ("not_last", i32), ("mix_self", i32), ("wait_ns", i64), ("gate", vp),
                ("ticket", vp), ("skipped", vp)]


class BarrierArgs(C.Structure):
    _fields_ = [("flags", vp * MAX_RANKS), ("epoch_ptr", vp), ("status", vp), ("rank", i32), ("world", i32),
                ("slot", i32), ("wait_ns", i64)]


_bound = {}


def fn(name):
    """The launcher `name`, with its signature declared."""
    if name not in _bound:
        from .. import _native
        _bound[name] = _native.register(name, SIGS[name])
    return _bound[name]
