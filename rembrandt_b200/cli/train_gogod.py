"""train-gogod: Go move prediction on 19 x 19 bit-plane positions, 361 classes (tools/train-gogod.rs: residual
network of a batch-normalised stem and five blocks, batch 256, constant step 0.1, no momentum, no weight decay,
display every 50 and validate every 1500 iterations). Positions come from a `.data` descriptor; without one,
seeded synthetic planes stand in for the game records."""
from ..models import zoo
from .common import base_parser, run_training


def main(argv=None):
    ap = base_parser(__doc__, batch=256, lr=0.1, momentum="zero", l2=0.0, iters=100, display_iters=50, valid_iters=0)
    ap.add_argument("--arch", choices=["resnet", "plain"], default="resnet",
                    help="resnet: the enabled network of the reference tool; plain: its commented-out 3x3 stack")
    ap.add_argument("--planes", type=int, default=32)
    ap.add_argument("--channels", type=int, default=128)
    ap.add_argument("--blocks", type=int, default=5)
    args = ap.parse_args(argv)
    if args.arch == "resnet":
        cfg = zoo.go_policy_resnet(args.planes, args.channels, args.blocks)
    else:
        cfg = zoo.go_policy_net(args.planes, args.channels, args.blocks + 1)
    return run_training(args, cfg)


if __name__ == "__main__":
    main()
