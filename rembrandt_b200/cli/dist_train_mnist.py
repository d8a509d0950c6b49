"""dist-train-mnist: the MNIST network trained data-parallel, one rank per GPU (tools/dist-train-mnist.rs: the
LeNet-style network of train-mnist with synchronous gradient averaging over all workers). Launch with
``python -m torch.distributed.run --nproc-per-node N -m rembrandt_b200.cli.dist_train_mnist``; with one process it
is train-mnist."""
from . import train_mnist


def main(argv=None):
    argv = list(argv) if argv is not None else None
    return train_mnist.main(argv)


if __name__ == "__main__":
    main()
