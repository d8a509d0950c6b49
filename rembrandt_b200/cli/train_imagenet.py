"""train-imagenet: AlexNet, NIN, VGG-A or ResNet-10/18/34 on ImageNet-shaped data (tools/train-imagenet.rs and the
examples/*.model descriptors). `--model-file` runs a .model descriptor instead of a built-in template."""
from ..models import descriptor, zoo
from ..optim.sgd import StepSizeSchedule
from .common import base_parser, run_training


def main(argv=None):
    ap = base_parser(__doc__, batch=64, lr=0.01, momentum="update", l2=5e-4, iters=100, display_iters=20)
    ap.add_argument("--model", default="alexnet",
                    choices=["alexnet", "nin", "vgg_a", "vgg_a_avgpool", "resnet10", "resnet18", "resnet20", "resnet34",
                             "resnet18_var",
                             "resnet34_var"])
    ap.add_argument("--model-file", default=None)
    args = ap.parse_args(argv)
    schedule = None
    if args.model_file:
        d = descriptor.load_model(args.model_file)
        cfg = d.config
        if d.opt is not None:
            schedule = d.opt.step_size
    elif args.model in ("alexnet", "nin"):
        cfg = getattr(zoo, args.model)(scale=1.0 / 255.0)
    elif args.model.endswith("_var"):
        cfg = getattr(zoo, args.model)()
    else:
        cfg = getattr(zoo, args.model)(mean=None)
    return run_training(args, cfg, schedule or StepSizeSchedule.decay(args.lr, 0.1, 200000))


if __name__ == "__main__":
    main()
