"""Operator configurations and the fluent sequential builder.

Counterpart of the reference's per-operator ``*OperatorConfig`` structs, its ``OperatorConfig`` tagged union
(src/operator/mod.rs:121-231), the enums next to it (``ActivationFunction``, ``ParamsInit``, ``PoolOperation``,
``OpPhase``, ``Regularization``; :233-297) and ``SequentialOperatorConfig`` with its ``.data3d().conv2d()...``
builder methods (src/operator/worker.rs:133-228).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple


class Act(enum.Enum):
    IDENTITY = "identity"
    RECT = "rect"
    LOGISTIC = "logistic"   # gen-3 of the reference declares these two without implementing them; gen-1 has them
    TANH = "tanh"
    BOUNDED_RECT = "bounded_rect"   # min(max(x, 0), bound): the gen-1 clipped ReLU (src/layer.rs:55)
    SCALED_LOGISTIC = "scaled_logistic"   # sigmoid(beta x): gen-2 ScaledSigmoid{beta} (src/layer_new.rs:164)

    @staticmethod
    def parse(s: str) -> "Act":
        s = s.lower()
        if s in ("relu", "rect"):
            return Act.RECT
        if s in ("identity", "none", "linear"):
            return Act.IDENTITY
        if s in ("sigmoid", "logistic"):
            return Act.LOGISTIC
        if s == "tanh":
            return Act.TANH
        if s in ("bounded_rect", "boundedrect"):
            return Act.BOUNDED_RECT
        if s in ("scaled_sigmoid", "scaled_logistic"):
            return Act.SCALED_LOGISTIC
        raise ValueError(f"unknown activation {s!r}")


# Default upper clip of Act.BOUNDED_RECT (the reference's kernel takes no bound argument and its source is not in
# the tree, so the value is this framework's choice) and default beta of Act.SCALED_LOGISTIC. An operator
# configuration's `act_param` overrides them.
ACT_BOUND = 6.0
ACT_BETA = 1.0


class OpPhase(enum.Enum):
    INFERENCE = 0
    TRAINING = 1


class OpCapability(enum.Enum):
    FORWARD = 0
    BACKWARD = 1


@dataclass
class ParamsInit:
    """kind: disabled | uniform (half_range) | normal (std) | xavier | kaiming_fwd"""
    kind: str = "disabled"
    half_range: float = 0.0
    std: float = 0.0
    mean: float = 0.0

    @staticmethod
    def uniform(half_range):
        return ParamsInit("uniform", half_range=half_range)

    @staticmethod
    def normal(std, mean=0.0):
        return ParamsInit("normal", std=std, mean=mean)

    @staticmethod
    def xavier():
        return ParamsInit("xavier")

    @staticmethod
    def kaiming():
        return ParamsInit("kaiming_fwd")


class PoolKind(enum.Enum):
    MAX = "max"
    AVERAGE = "average"


@dataclass
class BNormMovingAverage:
    """Running-statistics factor: cumulative 1/(1+t) or exponential f (1.0 at t = 0); conv.rs:52-73."""
    kind: str = "exponential"
    factor: float = 0.1

    def at_iter(self, t: int) -> float:
        if self.kind == "cumulative":
            return 1.0 / (1.0 + t)
        return 1.0 if t == 0 else self.factor


# ---------------------------------------------------------------------------------------- preprocessing
@dataclass
class Preproc:
    """One stage of the input operator's preprocessing chain (src/operator/mod.rs:491-519).

    kind: crop (crop_width, crop_height, pad) | flip_x | subtract_mean (mean_path or mean array, normalize) |
    pca_noise (std, eigenvalues, eigenvectors) | scale_bicubic (lower, upper; variable-size input only)
    """
    kind: str
    crop_width: int = 0
    crop_height: int = 0
    pad: int = 0
    mean_path: Optional[str] = None
    mean: Optional[object] = None
    normalize: bool = False
    std: float = 0.0
    eigenvalues: Sequence[float] = ()
    eigenvectors: Sequence[float] = ()
    lower: int = 0
    upper: int = 0


@dataclass
class Data3dCfg:
    in_dims: Tuple[int, int, int]            # (W, H, C) as in the reference
    normalize: bool = False                  # divide bytes by 255
    preprocs: List[Preproc] = field(default_factory=list)
    per_batch_draws: bool = False            # one crop offset / flip coin per batch (reference behaviour)
    scale: Optional[float] = None            # overrides the 1/255 factor when set
    variable_size: bool = False              # VarData3d: per-sample source shapes (src/operator/input.rs)
    max_dims: Optional[Tuple[int, int, int]] = None   # largest (W, H, C) a variable-size sample may have
    channel_mean: Optional[Sequence[float]] = None    # variable-size input: per-channel mean (after scaling)


class ConvBackend(enum.Enum):
    """Which kernels a convolution runs on. The reference's enum of the same name picks a cuDNN algorithm
    (implicit precomputed GEMM or tiled FFT, src/layer_new.rs:177,837-838); here the choice is between the tcgen05
    implicit GEMM and the plain CUDA-core kernels kept as its on-device cross-check."""
    TENSOR_CORE = "tensor_core"
    DIRECT = "direct"


@dataclass
class Conv2dCfg:
    conv_size: int
    conv_stride: int
    conv_pad: int
    out_channels: int
    act: Act = Act.RECT
    init_weights: ParamsInit = field(default_factory=lambda: ParamsInit.kaiming())
    bias: bool = True
    backend: ConvBackend = ConvBackend.TENSOR_CORE
    act_param: Optional[float] = None


@dataclass
class ResConv2dCfg:
    """Residual convolution without normalisation: out = act(conv(x) + b + x), stride 1, "same" padding, as many output
    as input channels (ResidualConv2dLayer of the second layer generation, src/layer_new.rs:1179-1418)."""
    conv_size: int = 3
    act: Act = Act.RECT
    init_weights: ParamsInit = field(default_factory=lambda: ParamsInit.kaiming())
    bias: bool = True
    act_param: Optional[float] = None


@dataclass
class AffineCfg:
    out_channels: int
    act: Act = Act.IDENTITY
    init_weights: ParamsInit = field(default_factory=lambda: ParamsInit.xavier())
    bias: bool = True
    act_param: Optional[float] = None


@dataclass
class MimicAffineCfg:
    """Low-rank fully connected block of the first layer generation (MimicAffineLayerConfig, src/layer.rs:817-824):
    in -> `bottleneck_rank` (no bias, no activation) -> `hidden_channels` (no bias, `hidden_act`) -> `out_channels`
    (bias). It is a macro: `SequentialOperatorConfig.mimic_affine` expands it into three affine operators."""
    bottleneck_rank: int
    hidden_channels: int
    out_channels: int
    hidden_act: Act = Act.RECT
    init_weights: ParamsInit = field(default_factory=lambda: ParamsInit.xavier())


@dataclass
class Pool2dCfg:
    pool_size: int
    pool_stride: int
    pool_pad: int = 0
    kind: PoolKind = PoolKind.MAX
    ceil_mode: bool = False                  # gen-3 floors (mod.rs:2022-2027), gen-1 / .model files ceil
    act: Act = Act.IDENTITY


@dataclass
class LrnCfg:
    cross_size: int = 5
    scale: float = 1e-4                      # alpha, applied to the plain sum of squares over the window
    power: float = 0.75
    min_div: float = 2.0
    alpha_div_n: bool = False                # Caffe / torch divide alpha by the window size


@dataclass
class DropoutCfg:
    drop_ratio: float = 0.5


@dataclass
class BNormConv2dCfg:
    conv_size: int
    conv_stride: int
    conv_pad: int
    out_channels: int
    act: Act = Act.RECT
    init_weights: ParamsInit = field(default_factory=lambda: ParamsInit.kaiming())
    bnorm_mov_avg: BNormMovingAverage = field(default_factory=BNormMovingAverage)
    bnorm_epsilon: float = 1e-5


@dataclass
class StackResConv2dCfg:
    """Identity basic block: relu(x + bn(conv3x3(relu(bn(conv3x3(x))))))."""
    init_weights: ParamsInit = field(default_factory=lambda: ParamsInit.kaiming())
    bnorm_mov_avg: BNormMovingAverage = field(default_factory=BNormMovingAverage)
    bnorm_epsilon: float = 1e-5


@dataclass
class ProjStackResConv2dCfg:
    """Projection basic block; stride 2 when the output is half the input size, else 1."""
    out_channels: int
    out_hw: Optional[int] = None             # None: halve the spatial size when channels change
    init_weights: ParamsInit = field(default_factory=lambda: ParamsInit.kaiming())
    bnorm_mov_avg: BNormMovingAverage = field(default_factory=BNormMovingAverage)
    bnorm_epsilon: float = 1e-5


@dataclass
class BotResConv2dCfg:
    """Bottleneck residual block (configuration only, as in the reference: conv.rs:3854-3886)."""
    bottleneck_channels: int = 0
    out_channels: int = 0


@dataclass
class SoftmaxKLLossCfg:
    num_categories: int


@dataclass
class PointwiseLossCfg:
    """Logistic (binary cross-entropy on logits) or L2 head over `num_outputs` outputs with float targets."""
    num_outputs: int = 1
    kind: str = "logistic"       # "logistic" | "l2"


@dataclass
class MultiSoftmaxKLLossCfg:
    """`num_heads` softmax heads of `num_categories` each (look-ahead targets, src/layer_new.rs:2969-3118)."""
    num_categories: int
    num_heads: int = 1


@dataclass
class MarginalizedSoftmaxIndLossCfg:
    num_categories: int


@dataclass
class CategoricalObjLossCfg:
    """Categorical heads of the second layer generation other than softmax + cross-entropy (src/layer_new.rs:2136
    SoftmaxIndicatorLossLayer, :2637 AntilogisticKLLossLayer, :2859 AntilogisticIndicatorLossLayer):
    kind = "softmax_ind" | "antilogistic_kl" | "antilogistic_ind"."""
    num_categories: int
    kind: str = "softmax_ind"


@dataclass
class SplitCfg:
    """Fan-out marker for the graph container: the activation is shared, branch deltas are summed."""
    num_out_arms: int = 2


@dataclass
class JoinCfg:
    """Fan-in for the graph container: the arms (same shape) are summed; every arm receives the output's delta."""
    num_in_arms: int = 2


OpCfg = object


@dataclass
class NamedOp:
    name: str
    cfg: OpCfg


class SequentialOperatorConfig:
    """input operator -> hidden operators -> loss operator, built fluently."""

    def __init__(self):
        self.input_op: Optional[NamedOp] = None
        self.hidden_ops: List[NamedOp] = []
        self.loss_op: Optional[NamedOp] = None

    def _name(self, name, prefix):
        return name if name else f"{prefix}{len(self.hidden_ops) + 1}"

    def data3d(self, cfg: Data3dCfg, name="data"):
        self.input_op = NamedOp(name, cfg)
        return self

    def var_data3d(self, cfg: Data3dCfg, name="data"):
        cfg.variable_size = True
        self.input_op = NamedOp(name, cfg)
        return self

    def conv2d(self, cfg: Conv2dCfg, name=None):
        self.hidden_ops.append(NamedOp(self._name(name, "conv"), cfg))
        return self

    def res_conv2d(self, cfg: ResConv2dCfg, name=None):
        self.hidden_ops.append(NamedOp(self._name(name, "resconv"), cfg))
        return self

    def bnorm_conv2d(self, cfg: BNormConv2dCfg, name=None):
        self.hidden_ops.append(NamedOp(self._name(name, "bnconv"), cfg))
        return self

    def stack_res_conv2d(self, cfg: StackResConv2dCfg, name=None):
        self.hidden_ops.append(NamedOp(self._name(name, "res"), cfg))
        return self

    def proj_stack_res_conv2d(self, cfg: ProjStackResConv2dCfg, name=None):
        self.hidden_ops.append(NamedOp(self._name(name, "projres"), cfg))
        return self

    def bot_res_conv2d(self, cfg, name=None):
        raise NotImplementedError("bottleneck residual blocks are configuration-only, as in the reference "
                                  "(src/operator/worker.rs:204-212)")

    def pool2d(self, cfg: Pool2dCfg, name=None):
        self.hidden_ops.append(NamedOp(self._name(name, "pool"), cfg))
        return self

    def lrn(self, cfg: LrnCfg, name=None):
        self.hidden_ops.append(NamedOp(self._name(name, "lrn"), cfg))
        return self

    def dropout(self, cfg: DropoutCfg, name=None):
        self.hidden_ops.append(NamedOp(self._name(name, "drop"), cfg))
        return self

    def affine(self, cfg: AffineCfg, name=None):
        self.hidden_ops.append(NamedOp(self._name(name, "fc"), cfg))
        return self

    def mimic_affine(self, cfg: MimicAffineCfg, name=None):
        base = self._name(name, "mimic")
        init = cfg.init_weights
        self.affine(AffineCfg(cfg.bottleneck_rank, Act.IDENTITY, init, bias=False), base + ".down")
        self.affine(AffineCfg(cfg.hidden_channels, cfg.hidden_act, init, bias=False), base + ".up")
        return self.affine(AffineCfg(cfg.out_channels, Act.IDENTITY, init), base + ".out")

    def softmax_kl_loss(self, cfg: SoftmaxKLLossCfg, name="loss"):
        self.loss_op = NamedOp(name, cfg)
        return self

    def marginalized_softmax_ind_loss(self, cfg: MarginalizedSoftmaxIndLossCfg, name="loss"):
        self.loss_op = NamedOp(name, cfg)
        return self

    def categorical_obj_loss(self, cfg: "CategoricalObjLossCfg", name="loss"):
        self.loss_op = NamedOp(name, cfg)
        return self

    def pointwise_loss(self, cfg: "PointwiseLossCfg", name="loss"):
        self.loss_op = NamedOp(name, cfg)
        return self

    def multi_softmax_kl_loss(self, cfg: "MultiSoftmaxKLLossCfg", name="loss"):
        self.loss_op = NamedOp(name, cfg)
        return self

    def validate(self):
        if self.input_op is None or self.loss_op is None:
            raise ValueError("a sequential configuration needs an input and a loss operator")
        return self


class GraphOperatorConfig:
    """A directed acyclic graph of named operators (src/operator/worker.rs:479-596).

    Every node names its inputs. `linearize()` inserts a Split node wherever an output feeds more than one consumer
    (as the reference's builder does) and orders the nodes by a depth-first topological sort that starts from the
    loss; the network container then runs them forward in that order and backward in the reverse order.
    The reference stops at the sorted configuration (its `into_worker` is unimplemented); here the graph runs.
    """

    def __init__(self):
        self.nodes = {}          # name -> (cfg, [input names]) in insertion order
        self.input_name: Optional[str] = None
        self.loss_name: Optional[str] = None

    def input(self, name: str, cfg: Data3dCfg):
        self.nodes[name] = (cfg, [])
        self.input_name = name
        return self

    def op(self, name: str, cfg: OpCfg, inputs):
        if name in self.nodes:
            raise ValueError(f"duplicate operator name {name!r}")
        self.nodes[name] = (cfg, [inputs] if isinstance(inputs, str) else list(inputs))
        return self

    def loss(self, name: str, cfg: OpCfg, inp: str):
        self.op(name, cfg, [inp])
        self.loss_name = name
        return self

    def validate(self):
        if self.input_name is None or self.loss_name is None:
            raise ValueError("a graph configuration needs an input and a loss operator")
        for name, (cfg, ins) in self.nodes.items():
            for i in ins:
                if i not in self.nodes:
                    raise ValueError(f"operator {name!r} reads the unknown operator {i!r}")
            if isinstance(cfg, JoinCfg) and len(ins) != cfg.num_in_arms:
                raise ValueError(f"join {name!r} expects {cfg.num_in_arms} inputs, has {len(ins)}")
            if not isinstance(cfg, JoinCfg) and name != self.input_name and len(ins) != 1:
                raise ValueError(f"operator {name!r} needs exactly one input")
        return self

    def linearize(self):
        """[(name, cfg, [producer keys])] in execution order. A producer key is an operator name, or
        "<split name>:<arm>" for one arm of an inserted Split."""
        self.validate()
        consumers = {}
        for name, (_cfg, ins) in self.nodes.items():
            for i in ins:
                consumers.setdefault(i, []).append(name)
        nodes = {}
        rename = {}               # (consumer, producer) -> producer key
        for name, (cfg, ins) in self.nodes.items():
            nodes[name] = [cfg, list(ins)]
        for prod, cons in consumers.items():
            if len(cons) > 1:
                split = f"{prod}__split"
                nodes[split] = [SplitCfg(len(cons)), [prod]]
                for arm, c in enumerate(cons):
                    rename[(c, prod)] = f"{split}:{arm}"
        for name, (_cfg, ins) in nodes.items():
            if not isinstance(_cfg, SplitCfg):
                nodes[name][1] = [rename.get((name, i), i) for i in ins]
        order, state = [], {}

        def visit(name):
            if state.get(name) == 2:
                return
            if state.get(name) == 1:
                raise ValueError(f"the operator graph has a cycle through {name!r}")
            state[name] = 1
            for key in nodes[name][1]:
                visit(key.split(":")[0])
            state[name] = 2
            order.append(name)

        visit(self.loss_name)
        return [(n, nodes[n][0], nodes[n][1]) for n in order]
