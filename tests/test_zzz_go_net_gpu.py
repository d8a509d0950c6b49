"""Go move-prediction networks (361 logits on a 19 x 19 x 1 plane) on the device against the CPU reference path."""
import pytest
import torch

from rembrandt_b200.models import zoo
from rembrandt_b200.models.net import Net
from rembrandt_b200.ops import native_ops as K

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("template", ["go_policy_net", "go_policy_resnet"])
def test_go_network_matches_reference_path(template):
    batch = 8
    make = lambda: (zoo.go_policy_net(8, 32, 3) if template == "go_policy_net" else zoo.go_policy_resnet(8, 32, 2))
    g = Net(make(), batch, device="cuda", seed=(3, 4))
    c = Net(make(), batch, device="cpu", seed=(3, 4))
    with torch.no_grad():
        c.params.copy_(g.params16.float().cpu())
    torch.manual_seed(0)
    x = (torch.rand(batch, 8, 19, 19) < 0.3).to(torch.uint8) * 255
    y = torch.randint(0, 361, (batch,))
    g.load_batch(x.cuda(), y.cuda().int())
    c.load_batch(x, y)
    for n in (g, c):
        n.forward(True)
        n.backward()
    torch.cuda.synchronize()
    assert K.read_status() == 0
    gl, _ = g.read_stats()
    cl, _ = c.read_stats()
    assert abs(gl - cl) < 3e-2 * max(1.0, abs(cl)), (gl, cl)
    gg, cg = g.grads.cpu(), c.grads
    biggest = max(float(cg[s.offset: s.offset + s.numel].norm()) for s in g.segs)
    for seg in g.segs:
        a, b = gg[seg.offset: seg.offset + seg.numel], cg[seg.offset: seg.offset + seg.numel]
        if float(b.norm()) < 1e-3 * biggest:
            continue    # the bias behind the one-channel move plane: its gradient is a sum of deltas that cancels
        # the 361-way softmax over one plane sums deltas that nearly cancel, so bf16 rounding noise is large here;
        # it is unbiased, so the component along the reference gradient stays at 1
        rel = float((a - b).norm() / b.norm())
        along = float((a * b).sum() / (b * b).sum())
        assert rel < 0.35, f"{seg.name}: relative error {rel:.4g}"
        assert abs(along - 1.0) < 0.1, f"{seg.name}: component along the reference gradient {along:.4g}"
    picks = g.loss_op.sample_categories(temperature=0.5)
    assert picks.shape == (batch,) and int(picks.max()) < 361
