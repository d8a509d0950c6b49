"""train-mnist: LeNet-style network on MNIST-shaped data (tools/train-mnist.rs: conv 20/50 + fc 500, step 0.01,
Nesterov 0.9). `--data examples/mnist.data` trains on the real IDX files; without it, seeded synthetic digits."""
from ..models import zoo
from .common import base_parser, run_training


def main(argv=None, doc=None, **defaults):
    """`defaults` override the parser's defaults (the data-parallel tool has its own step size and momentum)."""
    base = dict(batch=64, lr=0.01, momentum="nesterov", l2=5e-4, iters=300, valid_iters=4, checkpoint_iters=0)
    base.update(defaults)
    ap = base_parser(doc or __doc__, **base)
    ap.add_argument("--pad", type=int, default=2, help="conv padding (2 as in the reference tool, 0 for the 800-input fc)")
    ap.add_argument("--model", choices=["lenet", "fc1", "fc2"], default="lenet")
    args = ap.parse_args(argv)
    cfg = {"lenet": lambda: zoo.lenet(pad=args.pad), "fc1": zoo.mnist_fc1, "fc2": zoo.mnist_fc2}[args.model]()
    return run_training(args, cfg)


if __name__ == "__main__":
    main()
