"""run-rembrandt: train the network of a `.model` descriptor on the splits of a `.data` descriptor -- the
descriptor-driven driver of the reference's first generation (tools/run-rembrandt.rs:24-122 opens
examples/mnist_lenet.model and examples/mnist.data, trains on the "train" split and evaluates on "test").
The optimizer section of the model file, when present, provides the step-size schedule."""
from ..data import open_split
from ..data.datasets import load_data
from ..models import descriptor
from .common import base_parser, run_training


def main(argv=None):
    ap = base_parser(__doc__, batch=64, lr=0.01, momentum="update", l2=5e-4, iters=200, display_iters=50,
                     valid_iters=4)
    ap.add_argument("--model-file", default="examples/mnist_lenet.model")
    first, _ = ap.parse_known_args(argv)
    d = descriptor.load_model(first.model_file)
    schedule = None
    if d.opt is not None:
        # the optimizer section of the model file provides the defaults; flags on the command line still win
        schedule = d.opt.step_size
        ap.set_defaults(minibatch=d.opt.minibatch_size, mu=d.opt.mu, l2=d.opt.l2_reg_coef, lr=d.opt.step_size.at_iter(0))
    args = ap.parse_args(argv)
    if args.minibatch and args.minibatch % args.batch:
        args.batch = args.minibatch if args.minibatch < args.batch else args.batch
        args.minibatch = args.minibatch // args.batch * args.batch
    source = valid = None
    if args.data:
        splits = load_data(args.data)
        if "train" not in splits:
            raise SystemExit(f"{args.data}: missing train data source")
        held_out = next((s for s in ("valid", "test") if s in splits), None)   # gen-1 files call the split "test"
        source = open_split(splits["train"])         # a synthetic split is given the model's shape by run_training
        valid = open_split(splits[held_out]) if held_out and args.valid_iters else None
    return run_training(args, d.config, schedule, source=source, valid_source=valid)


if __name__ == "__main__":
    main()
