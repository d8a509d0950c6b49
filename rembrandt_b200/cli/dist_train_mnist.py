"""dist-train-mnist: the MNIST network trained data-parallel, one rank per GPU (tools/dist-train-mnist.rs: the
LeNet-style network of train-mnist under the distributed worker, constant step 0.001 and no momentum -- the
reference keeps its momentum variants commented out there -- gradients averaged over all workers before the step).

    python -m torch.distributed.run --nproc-per-node N -m rembrandt_b200.cli.dist_train_mnist [--comm gossip_p2p ...]

`--comm` selects any exchange backend (default: the fused all-reduce + SGD kernels on GPUs, library all-reduce on CPU
ranks); with one process it trains like train-mnist with these settings."""
from . import train_mnist


def main(argv=None):
    return train_mnist.main(argv, doc=__doc__, lr=0.001, momentum="zero", comm="auto")


if __name__ == "__main__":
    main()
