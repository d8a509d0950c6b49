"""Graph container: automatic Split insertion, topological order, Split / Join operators."""
import pytest
import torch
import torch.nn.functional as F

from rembrandt_b200.models import config as C
from rembrandt_b200.models.net import Net
from rembrandt_b200.models.operators import JoinOp, SplitOp


def residual_graph(hw=12):
    """data -> conv1 (ReLU) -> [conv2a -> conv2b] + identity -> join -> pool -> fc -> loss."""
    k = C.ParamsInit.kaiming()
    g = C.GraphOperatorConfig()
    g.input("data", C.Data3dCfg((hw, hw, 3), normalize=True))
    g.op("conv1", C.Conv2dCfg(3, 1, 1, 32, C.Act.RECT, k), "data")
    g.op("conv2a", C.Conv2dCfg(3, 1, 1, 32, C.Act.RECT, k), "conv1")
    g.op("conv2b", C.Conv2dCfg(3, 1, 1, 32, C.Act.IDENTITY, k), "conv2a")
    g.op("sum", C.JoinCfg(2), ["conv2b", "conv1"])
    g.op("pool", C.Pool2dCfg(2, 2, 0, C.PoolKind.AVERAGE, act=C.Act.RECT), "sum")
    g.op("fc", C.AffineCfg(10, C.Act.IDENTITY, C.ParamsInit.xavier()), "pool")
    g.loss("loss", C.SoftmaxKLLossCfg(10), "fc")
    return g


def test_linearize_inserts_split_and_orders_topologically():
    order = residual_graph().linearize()
    names = [n for n, _, _ in order]
    assert names[0] == "data" and names[-1] == "loss"
    assert "conv1__split" in names
    pos = {n: i for i, n in enumerate(names)}
    for n, _cfg, ins in order:
        for key in ins:
            assert pos[key.split(":")[0]] < pos[n]
    by = {n: ins for n, _, ins in order}
    assert sorted(by["conv2a"] + [by["sum"][1]]) == ["conv1__split:0", "conv1__split:1"]
    assert by["sum"][0] == "conv2b"


def test_cycle_and_unknown_input_are_rejected():
    g = C.GraphOperatorConfig().input("data", C.Data3dCfg((8, 8, 3)))
    g.op("a", C.Pool2dCfg(1, 1), "b").op("b", C.Pool2dCfg(1, 1), "a")
    g.loss("loss", C.SoftmaxKLLossCfg(10), "b")
    with pytest.raises(ValueError, match="cycle"):
        g.linearize()
    g2 = C.GraphOperatorConfig().input("data", C.Data3dCfg((8, 8, 3)))
    g2.op("a", C.Pool2dCfg(1, 1), "nope").loss("loss", C.SoftmaxKLLossCfg(10), "a")
    with pytest.raises(ValueError, match="unknown"):
        g2.linearize()


def test_graph_net_cpu_matches_manual_torch():
    net = Net(residual_graph(), 4, device="cpu", seed=(3, 4))
    kinds = [type(o) for o in net.ops]
    assert SplitOp in kinds and JoinOp in kinds
    torch.manual_seed(0)
    x = torch.randint(0, 256, (4, 3, 12, 12), dtype=torch.uint8)
    y = torch.randint(0, 10, (4,))
    net.load_batch(x, y)
    net.forward(True)
    net.backward()
    loss = net.read_stats()[0]
    ops = {o.name: o for o in net.ops}

    # rebuild the forward pass with plain torch ops through each operator's own reference function, wiring the
    # graph by hand: this checks the container's routing, not the operators' maths
    xin = ops["data"].ref_forward(x, True, 0)
    a1 = ops["conv1"].ref_forward(xin, True, 0)
    b = ops["conv2b"].ref_forward(ops["conv2a"].ref_forward(a1, True, 0), True, 0)
    s = b + a1
    logits = ops["fc"].ref_forward(ops["pool"].ref_forward(s, True, 0), True, 0)
    manual = F.cross_entropy(logits.flatten(1), y, reduction="sum") / 4
    assert abs(float(manual.detach()) - loss) < 1e-5 * max(1.0, abs(loss))
    assert float(net.grads.abs().sum()) > 0


@pytest.mark.gpu
def test_graph_net_gpu_matches_cpu_path():
    from rembrandt_b200.ops import native_ops as K
    g = Net(residual_graph(), 6, device="cuda", seed=(3, 4))
    c = Net(residual_graph(), 6, device="cpu", seed=(3, 4))
    with torch.no_grad():
        c.params.copy_(g.params16.float().cpu())
    torch.manual_seed(0)
    x = torch.randint(0, 256, (6, 3, 12, 12), dtype=torch.uint8)
    y = torch.randint(0, 10, (6,))
    g.load_batch(x.cuda(), y.cuda().int())
    c.load_batch(x, y)
    for n in (g, c):
        n.forward(True)
        n.backward()
    torch.cuda.synchronize()
    assert K.read_status() == 0
    gl, cl = g.read_stats()[0], c.read_stats()[0]
    assert abs(gl - cl) < 3e-2 * max(1.0, abs(cl)), (gl, cl)
    gg, cg = g.grads.cpu(), c.grads
    for seg in g.segs:
        a = gg[seg.offset: seg.offset + seg.numel]
        b = cg[seg.offset: seg.offset + seg.numel]
        rel = float((a - b).norm() / b.norm().clamp_min(1e-12))
        assert rel < 8e-2, f"{seg.name}: relative error {rel:.4g}"
