"""Readers for the reference's TOML descriptors.

``.model`` files (examples/mnist_lenet.model, imagenet_alexnet.model, imagenet_nin.model): ``[[layer]]``
tables with ``name``/``names``, optional ``input``/``inputs`` and a ``type`` in {data, fully_conn, conv2d, pool,
local_res_norm, dropout, softmax_loss}, plus an ``[opt]`` table. The reference's own parser
(src/config.rs:11-265) rejects the shipped AlexNet file; this one accepts all three as shipped:

* a missing ``type`` is inferred from the keys (``pool_size`` -> pool, ``out_channels`` without ``conv_size``
  -> fully_conn, ...);
* ``act_func = "relu"`` is ``"rect"``; ``pool_kind`` defaults to ``"max"``; ``act_func`` on a pool layer is honoured;
* ``names = [a, b]`` towers are merged into one layer with the summed channel count (the ungrouped network:
  the reference's parser also only instantiates duplicate layers, no device placement exists);
* pooling output sizes round up, as in the gen-1 layer this format belongs to (src/layer.rs:1741-1747);
* ``[opt]`` is read (the reference never reads it) into an ``SgdOptConfig``.

``.data`` files (examples/*.data): ``[dataset.<split>]`` tables with ``source``, ``data_path``, ``labels_path``,
``mean_path``, ``normalize`` (src/data_new.rs:296-342).
"""
from __future__ import annotations

import tomllib
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from ..optim.sgd import Momentum, SgdOptConfig, StepSizeSchedule
from . import config as C


class DescriptorError(ValueError):
    pass


def _infer_type(layer: dict) -> str:
    if "type" in layer:
        return layer["type"]
    if "pool_size" in layer:
        return "pool"
    if "conv_size" in layer:
        return "conv2d"
    if "cross_size" in layer:
        return "local_res_norm"
    if "drop_ratio" in layer:
        return "dropout"
    if "num_categories" in layer:
        return "softmax_loss"
    if "raw_width" in layer:
        return "data"
    if "out_channels" in layer:
        return "fully_conn"
    raise DescriptorError(f"cannot infer the type of layer {layer.get('name') or layer.get('names')}")


def _init(layer: dict) -> C.ParamsInit:
    iw = layer.get("init_weights")
    if not iw:
        return C.ParamsInit.normal(0.01)
    kind = iw.get("kind", "normal")
    if kind == "normal":
        return C.ParamsInit.normal(float(iw.get("std", 0.01)), float(iw.get("mean", 0.0)))
    if kind == "uniform":
        return C.ParamsInit.uniform(float(iw.get("half_range", 0.01)))
    if kind == "xavier":
        return C.ParamsInit.xavier()
    if kind in ("kaiming", "kaiming_fwd"):
        return C.ParamsInit.kaiming()
    raise DescriptorError(f"unknown init_weights kind {kind!r}")


@dataclass
class ModelDescriptor:
    config: C.SequentialOperatorConfig
    opt: Optional[SgdOptConfig]
    layer_names: List[str] = field(default_factory=list)
    raw_opt: Dict = field(default_factory=dict)


def parse_model(text: str, use_crop: bool = True) -> ModelDescriptor:
    doc = tomllib.loads(text)
    layers = doc.get("layer")
    if not layers:
        raise DescriptorError("no [[layer]] tables")
    cfg = C.SequentialOperatorConfig()
    names = []
    produced = {}     # layer name -> index of the merged layer that produces it
    for idx, layer in enumerate(layers):
        lnames = layer.get("names") or [layer.get("name")]
        if not lnames or lnames[0] is None:
            raise DescriptorError(f"layer {idx} has no name")
        towers = len(lnames)
        name = lnames[0][:-1] if towers > 1 and lnames[0][-1:] in "ab" else lnames[0]
        inputs = layer.get("inputs") or ([layer["input"]] if "input" in layer else [])
        for i in inputs:
            if i not in produced:
                raise DescriptorError(f"layer {name!r} reads unknown layer {i!r}")
            if produced[i] != len(names) - 1:
                raise DescriptorError(f"layer {name!r}: only chains are supported, {i!r} is not the previous layer")
        kind = _infer_type(layer)
        if kind == "data":
            rw, rh = int(layer["raw_width"]), int(layer["raw_height"])
            cw, ch = int(layer.get("crop_width", rw)), int(layer.get("crop_height", rh))
            pre = []
            if use_crop and (cw, ch) != (rw, rh):
                pre = [C.Preproc("flip_x"), C.Preproc("crop", crop_width=cw, crop_height=ch)]
            src = (rw, rh) if pre else (cw, ch)
            cfg.data3d(C.Data3dCfg((src[0], src[1], int(layer["channels"])), normalize=bool(layer.get("normalize", False)),
                                   preprocs=pre), name)
        elif kind == "conv2d":
            cfg.conv2d(C.Conv2dCfg(int(layer["conv_size"]), int(layer.get("conv_stride", 1)),
                                   int(layer.get("conv_pad", 0)), towers * int(layer["out_channels"]),
                                   C.Act.parse(layer.get("act_func", "identity")), _init(layer)), name)
        elif kind == "fully_conn":
            cfg.affine(C.AffineCfg(towers * int(layer["out_channels"]), C.Act.parse(layer.get("act_func", "identity")),
                                   _init(layer)), name)
        elif kind == "pool":
            pk = layer.get("pool_kind", "max")
            if pk not in ("max", "average"):
                raise DescriptorError(f"unknown pool_kind {pk!r}")
            cfg.pool2d(C.Pool2dCfg(int(layer["pool_size"]), int(layer.get("pool_stride", 1)),
                                   int(layer.get("pool_pad", 0)), C.PoolKind(pk), ceil_mode=True,
                                   act=C.Act.parse(layer.get("act_func", "identity"))), name)
        elif kind == "local_res_norm":
            cfg.lrn(C.LrnCfg(int(layer.get("cross_size", 5)), float(layer.get("scale", 1e-4)),
                             float(layer.get("power", 0.75)), float(layer.get("min_div", 2.0))), name)
        elif kind == "dropout":
            cfg.dropout(C.DropoutCfg(float(layer["drop_ratio"])), name)
        elif kind == "softmax_loss":
            cfg.softmax_kl_loss(C.SoftmaxKLLossCfg(int(layer["num_categories"])), name)
        else:
            raise DescriptorError(f"unknown layer type {kind!r}")
        names.append(name)
        for ln in lnames:
            produced[ln] = len(names) - 1
    cfg.validate()
    raw_opt = doc.get("opt", {})
    return ModelDescriptor(cfg, parse_opt(raw_opt) if raw_opt else None, names, raw_opt)


def parse_opt(opt: dict) -> SgdOptConfig:
    step0 = float(opt.get("init_step_size", 0.01))
    mu = float(opt.get("momentum", 0.0))
    return SgdOptConfig(
        minibatch_size=int(opt.get("minibatch_size", 64)),
        step_size=StepSizeSchedule.from_annealing_policy(step0, opt.get("annealing_policy")),
        momentum=Momentum.UPDATE if mu > 0 else Momentum.ZERO,
        mu=mu,
        l2_reg_coef=float(opt.get("l2_reg_coef", 0.0)),
        max_iters=int(opt.get("max_iters", 0)),
        display_iters=int(opt.get("display_interval", 100)),
    )


def load_model(path: str, **kw) -> ModelDescriptor:
    with open(path, "rb") as f:
        return parse_model(f.read().decode(), **kw)


@dataclass
class DatasetSplit:
    source: str
    data_path: Optional[str] = None
    labels_path: Optional[str] = None
    labels2_path: Optional[str] = None
    mean_path: Optional[str] = None
    normalize: bool = False
    # for `source = "synthetic"` (no counterpart in the reference): image size (W, H, C), classes, number of samples
    dims: Optional[tuple] = None
    num_classes: int = 10
    size: int = 10000


def parse_data(text: str) -> Dict[str, DatasetSplit]:
    doc = tomllib.loads(text)
    out = {}
    for split, tbl in doc.get("dataset", {}).items():
        if "source" not in tbl:
            raise DescriptorError(f"dataset.{split} has no source")
        out[split] = DatasetSplit(tbl["source"], tbl.get("data_path"), tbl.get("labels_path"),
                                  tbl.get("labels2_path"), tbl.get("mean_path"), bool(tbl.get("normalize", False)),
                                  tuple(tbl["dims"]) if "dims" in tbl else None, int(tbl.get("num_classes", 10)),
                                  int(tbl.get("size", 10000)))
    return out


def load_data(path: str) -> Dict[str, DatasetSplit]:
    with open(path, "rb") as f:
        return parse_data(f.read().decode())
