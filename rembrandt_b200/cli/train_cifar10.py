"""train-cifar10: the "krizh26" convnet (74 % / 76 % with preprocessing in the reference's notes) or ResNet-20
(tools/train-cifar10.rs). Mean subtraction, pad-4 random crop and flip run in the GPU input kernel."""
import numpy as np

from ..data import compute_mean, open_data_file
from ..models import zoo
from .common import base_parser, run_training


def main(argv=None):
    ap = base_parser(__doc__, batch=128, lr=0.01, momentum="nesterov", l2=5e-4, iters=300, valid_iters=4)
    ap.add_argument("--model", choices=["krizh26", "resnet20"], default="krizh26")
    ap.add_argument("--no-augment", action="store_true")
    args = ap.parse_args(argv)
    mean = None
    source = None
    if args.data:
        source = open_data_file(args.data, "train")
        mean = compute_mean(source, limit=10000)
    else:
        mean = np.full((3, 32, 32), 127.5, np.float32)
    fn = zoo.cifar_krizh26 if args.model == "krizh26" else zoo.resnet20_cifar
    return run_training(args, fn(augment=not args.no_augment, mean=mean), source=source)


if __name__ == "__main__":
    main()
