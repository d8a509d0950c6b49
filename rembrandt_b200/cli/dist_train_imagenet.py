"""dist-train-imagenet: data-parallel ImageNet training, one rank per GPU (tools/new-dist-train-imagenet.rs:
ResNet-18, batch 32, minibatch 128 per worker, step 0.1 -> 0.01 @ 18750 -> 0.001 @ 37500, Nesterov 0.9, L2 1e-4,
gradients synchronised then stepped; tools/dist-train-imagenet*.rs: the gossip / elastic variants).

    python -m torch.distributed.run --nproc-per-node 8 -m rembrandt_b200.cli.dist_train_imagenet --comm fused_allreduce_sgd
"""
from ..models import zoo
from ..optim.sgd import StepSizeSchedule
from .common import base_parser, run_training


def main(argv=None):
    ap = base_parser(__doc__, batch=32, minibatch=128, lr=0.1, momentum="nesterov", l2=1e-4, iters=100,
                     display_iters=20, comm="auto")
    ap.add_argument("--model", default="resnet18", choices=["alexnet", "nin", "vgg_a", "resnet18", "resnet34", "resnet18_var",
                                                           "resnet34_var"],
                    help="the *_var networks take images of any size (JPEG record stores): the configuration of the "
                         "reference's new-dist-train-imagenet")
    args = ap.parse_args(argv)
    if args.model in ("alexnet", "nin"):
        cfg = getattr(zoo, args.model)(scale=1.0 / 255.0)
    elif args.model.endswith("_var"):
        cfg = getattr(zoo, args.model)()
    else:
        cfg = getattr(zoo, args.model)(mean=None)
    sched = StepSizeSchedule.anneal2(args.lr, 18750, args.lr * 0.1, 37500, args.lr * 0.01)
    return run_training(args, cfg, sched)


if __name__ == "__main__":
    main()
